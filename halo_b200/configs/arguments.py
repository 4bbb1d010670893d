"""Argument dataclasses shared by every training script: model, data, optimisation, run and
parallelism (field names follow halo/configs/parallelism_arguments.py:22-288 and the Hugging Face
``TrainingArguments`` names the reference's recipes use)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

from halo_b200.config_validation import ConfigError
from halo_b200.parallel.config import ParallelismConfig


@dataclass
class ModelArguments:
    model_name_or_path: str = ""
    model_preset: str = ""                  # one of halo_b200.models.config.PRESETS when training from scratch
    init_from_scratch: bool = False
    torch_dtype: Literal["bfloat16", "float32"] = "bfloat16"
    trust_remote_code: bool = False
    freeze_patterns: list[str] | None = None      # regexes of parameter names to freeze
    train_only_patterns: list[str] | None = None  # or: train only what matches
    max_length: int = 0                     # 0 = the model's context window
    lowp_format: Literal["", "mxfp8", "mxfp4", "nvfp4"] = ""   # quantisation-aware training in a block-scaled format
    enable_mtp_head: bool = False           # train a multi-token-prediction head beside the next-token loss
    mtp_loss_weight: float = 0.3
    mtp_objective: Literal["joint", "detached"] = "joint"
    use_peft: bool = False                  # train low-rank adapters on frozen base weights
    lora_r: int = 16
    lora_alpha: float = 32.0
    lora_dropout: float = 0.0
    lora_target_modules: list[str] | str | None = None   # hub projection names, "experts.<name>" for routed experts, or "all-linear"
    adapter_path: str = ""                  # adapters to continue from (a directory holding adapter_model.safetensors)
    merge_adapters_on_save: bool = False    # save full weights with the adapters folded in instead of the adapters alone
    load_in_4bit: bool = False              # QLoRA: keep the frozen base matrices of the decoder layers as 4-bit blocks (needs use_peft)
    load_in_8bit: bool = False              # the same with one signed byte per value (int8 blocks of 64)
    bnb_4bit_quant_type: Literal["nf4", "fp4"] = "nf4"
    use_bnb_nested_quant: bool = False      # also store the block maxima in 8 bits
    reset_sinks: bool = True                # gpt-oss: neutralize the attention sinks for fine-tuning; false keeps them live and frozen
    train_sinks: bool = False               # gpt-oss: train the live sinks (needs reset_sinks: false and full fine-tuning)

    def lora_spec(self):
        from halo_b200.peft.lora import LoraSpec

        if not self.use_peft:
            return None
        kw = {"target_modules": self.lora_target_modules} if self.lora_target_modules else {}
        return LoraSpec(r=self.lora_r, alpha=self.lora_alpha, dropout=self.lora_dropout, **kw)

    def __post_init__(self):
        if self.use_peft and (self.freeze_patterns or self.train_only_patterns):
            raise ConfigError("use_peft freezes the base weights itself: drop freeze_patterns / train_only_patterns")
        if self.load_in_4bit and self.load_in_8bit:
            raise ConfigError("load_in_4bit and load_in_8bit: choose one storage for the frozen base")
        if self.load_in_8bit:
            self.load_in_4bit, self.bnb_4bit_quant_type = True, "int8"        # one code path: the storage kind differs
            if self.use_bnb_nested_quant:
                raise ConfigError("use_bnb_nested_quant is a 4-bit option")
        if self.load_in_4bit and not self.use_peft:
            raise ConfigError("load_in_4bit / load_in_8bit store frozen base weights: they need use_peft: true (QLoRA)")
        if self.load_in_4bit and self.merge_adapters_on_save:
            raise ConfigError("merge_adapters_on_save with load_in_4bit would fold the adapters into the rounded base: save the "
                              "adapters alone and merge them into the original checkpoint with the merge-adapter tool")
        if self.load_in_4bit and self.lowp_format:
            raise ConfigError("load_in_4bit and lowp_format both round the base weights: choose one")
        if self.train_sinks and self.reset_sinks:
            raise ConfigError("train_sinks: true contradicts reset_sinks: true - set reset_sinks: false alongside train_sinks")
        if self.train_sinks and self.use_peft:
            raise ConfigError("train_sinks needs full fine-tuning: with adapters keep the sinks live and frozen")
        if not self.use_peft and (self.adapter_path or self.merge_adapters_on_save):
            raise ConfigError("adapter_path / merge_adapters_on_save need use_peft: true")
        if not self.model_name_or_path and not self.model_preset:
            raise ConfigError("set model_name_or_path (a checkpoint directory) or model_preset (train from scratch)")
        if self.model_preset and not self.init_from_scratch and not self.model_name_or_path:
            self.init_from_scratch = True


@dataclass
class DataArguments:
    dataset_path: str = ""                  # directory or file of jsonl / parquet / preprocessed shards
    dataset_format: Literal["auto", "text", "messages", "prompt_completion", "preference", "tokens", "synthetic"] = "auto"
    eval_dataset_path: str = ""
    text_field: str = "text"
    packing: bool = True
    packed_row_length: int = 8192
    packing_strategy: Literal["sequential", "best_fit"] = "sequential"
    completion_only_loss: bool = False
    shuffle_seed: int = 0
    synthetic_vocab: int = 0
    doc_length_min: int = 256
    doc_length_max: int = 16384
    num_proc: int = 4
    cache_dir: str = ""                     # coordinated preprocessing cache (tokenise + pack once per filesystem scope); "" = every rank for itself


@dataclass
class TrainingArguments:
    output_dir: str = "runs/%Y%m%d-%H%M%S"
    overwrite_output_dir: bool = False
    max_steps: int = -1
    num_train_epochs: float = 1.0
    per_device_train_batch_size: int = 1     # packed rows per rank per micro-step
    gradient_accumulation_steps: int = 1
    learning_rate: float = 1e-5
    weight_decay: float = 0.01
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler_type: Literal["linear", "cosine", "constant", "constant_with_warmup"] = "cosine"
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    optim: Literal["adamw_bf16", "adamw_torch", "adamw_bf16_host_state", "adamw_q8", "flash_adamw", "muon"] = "adamw_bf16"
    bf16: bool = True
    gradient_checkpointing: bool = True
    gradient_checkpointing_plan: Literal["full", "auto"] = "full"   # auto: lighter policy where memory allows, planned after step 1
    use_fused_kernels: bool = True
    logging_steps: int = 1
    logging_nan_inf_filter: bool = False
    save_steps: int = 0
    save_total_limit: int = 0
    save_sharded_ep: bool = False
    eval_steps: int = 0
    seed: int = 42
    resume_from_checkpoint: str = ""         # "" = none, "auto" = newest complete checkpoint in output_dir
    allow_optimizer_warm_restart: bool = False
    max_consecutive_nonfinite_steps: int = 5
    report_to: str = "none"
    enable_torch_profiler: bool = False
    router_aux_loss_coef: float = 0.0
    moe_balancing: Literal["auto", "aux_loss", "bias_update", "none"] = "auto"

    def __post_init__(self):
        if self.gradient_accumulation_steps < 1 or self.per_device_train_batch_size < 1:
            raise ConfigError("per_device_train_batch_size and gradient_accumulation_steps must be >= 1")
        if self.learning_rate < 0 or self.max_grad_norm < 0:
            raise ConfigError("learning_rate and max_grad_norm must be >= 0")
        if not 0.0 <= self.warmup_ratio < 1.0:
            raise ConfigError("warmup_ratio must lie in [0, 1)")


@dataclass
class ParallelismArguments:
    expert_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1
    tensor_parallel_size: int = 1
    context_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    pipeline_microbatches: int = 0
    pipeline_schedule: Literal["1f1b", "gpipe"] = "1f1b"
    pipeline_split: list[int] | None = None
    ep_scope: Literal["auto", "node", "global"] = "auto"
    ep_buffer_backend: Literal["auto", "symmetric", "nccl", "elastic", "legacy"] = "auto"
    nvlink_domain_size: int = 0
    fsdp_reshard_after_forward: bool = False
    fsdp_reshard_after_backward: bool = True
    fsdp_defer_grad_sync: bool = False
    fsdp_shard_ep1_experts: bool = True
    use_hsdp: bool = False
    fp32_router: bool = False
    fp32_experts: bool = False
    fp32_non_ep_params: bool = False
    fp32_grad_reduce: bool = False
    bf16_optimizer: bool | None = None
    use_grouped_gemm: bool = True
    max_concurrent_loading: int | None = None
    ep_lazy_loading: bool = True

    def to_config(self, world_size: int = 0, global_rank: int = -1, init_from_scratch: bool = False) -> ParallelismConfig:
        return ParallelismConfig(
            world_size=world_size, global_rank=global_rank, nvlink_domain_size=self.nvlink_domain_size,
            ep_size=self.expert_parallel_size, expert_tp_size=self.expert_tensor_parallel_size,
            tp_size=self.tensor_parallel_size, cp_size=self.context_parallel_size, pp_size=self.pipeline_parallel_size,
            pp_schedule=self.pipeline_schedule, pp_microbatches=self.pipeline_microbatches, pp_split=self.pipeline_split,
            ep_scope=self.ep_scope, ep_buffer_backend=self.ep_buffer_backend, fp32_router=self.fp32_router,
            fp32_experts=self.fp32_experts, fp32_non_ep_params=self.fp32_non_ep_params,
            fp32_grad_reduce=self.fp32_grad_reduce, bf16_optimizer=self.bf16_optimizer,
            use_grouped_gemm=self.use_grouped_gemm, fsdp_reshard_after_forward=self.fsdp_reshard_after_forward,
            fsdp_reshard_after_backward=self.fsdp_reshard_after_backward, fsdp_defer_grad_sync=self.fsdp_defer_grad_sync,
            fsdp_shard_ep1_experts=self.fsdp_shard_ep1_experts, use_hsdp=self.use_hsdp,
            max_concurrent_loading=self.max_concurrent_loading, ep_lazy_loading=self.ep_lazy_loading,
            init_from_scratch=init_from_scratch)


# ---- per-method arguments ---------------------------------------------------------------------------
@dataclass
class SFTArguments:
    assistant_only_loss: bool = False
    dataset_text_field: str = "text"


@dataclass
class PreferenceArguments:
    preference_loss: Literal["dpo", "ipo", "kto", "smpo"] = "dpo"
    beta: float = 0.1
    label_smoothing: float = 0.0
    reference_free: bool = False
    kto_desirable_weight: float = 1.0
    kto_undesirable_weight: float = 1.0
    smpo_margin: float = 1.0
    sft_loss_weight: float = 0.0


@dataclass
class RewardArguments:
    center_rewards_coefficient: float = 0.0
    num_labels: int = 1


@dataclass
class EmbeddingArguments:
    temperature: float = 0.05
    pairs_per_row: int = 16
    pooling: Literal["last_token", "mean"] = "last_token"
    sentence_transformers_layout: bool = True      # write modules.json / 1_Pooling beside the final checkpoint


@dataclass
class DistillationArguments:
    teacher_model_name_or_path: str = ""
    distill_mode: Literal["teacher", "self", "sdpg"] = "teacher"
    temperature: float = 1.0
    kd_loss: Literal["forward_kl", "reverse_kl", "jsd"] = "forward_kl"
    kd_weight: float = 1.0
    ce_weight: float = 0.0
    top_k_logits: int = 0


@dataclass
class GRPOArguments:
    num_generations: int = 8
    max_prompt_length: int = 1024
    max_completion_length: int = 4096
    grpo_beta: float = 0.0                      # KL weight against the reference policy
    epsilon: float = 0.2
    epsilon_high: float = 0.28
    loss_type: Literal["grpo", "dapo", "dr_grpo", "bnpo"] = "dapo"
    scale_rewards: Literal["group", "batch", "none", "maxrl"] = "group"
    std_floor: float = 0.0
    importance_clip_max: float = 2.0
    token_budget: int = 65536
    num_iterations: int = 1
    sync_weights_every: int = 1
    trust_region_mask_fraction: float = 1.0
    is_geo_band_min: float | None = None        # keep a trajectory only if exp(mean log-ratio) lies in [min, max] (None = off)
    is_geo_band_max: float = 2.0
    is_veto_min: float | None = None            # drop a trajectory holding a token whose raw ratio falls below this (None = off)
    opsm_delta: float | None = None             # drop negative-advantage trajectories whose |mean log-ratio| exceeds this (None = off)
    zero_gradient_round_limit: int = 0
    sdpg_beta_base: float = 0.0                 # > 0: add beta(k) x on-policy self-distillation from a hinted pass of the policy
    sdpg_beta_warmup_steps: int = 0
    sdpg_beta_decay_steps: int = 0
    sdpg_loss: Literal["reverse_kl", "forward_kl", "jsd"] = "reverse_kl"
    sdpg_temperature: float = 1.0
    sdpg_answer_field: str = "answer"           # task-row field holding the gold answer the hint reveals
    sdpg_hint_template: str = "\n(The reference answer is: {answer})\n"
    opd_positive_advantage_only: bool = True    # distil only on rollouts the verifier preferred
    rollout_backend: Literal["in_process", "vllm", "sglang", "resident_copy"] = "resident_copy"
    rollout_gpus: int = 0
    rollout_server_url: str = ""                # vllm / sglang: http://host:port of the generation server
    rollout_served_model: str = ""              # the model name the server answers to (default: model_name_or_path)
    weight_sync_chunk_mb: int = 1024
    environment_type: str = ""                  # e.g. "qa", "code", "tool_qa": rollouts are episodes of this environment over the dataset's tasks
    environment_options: dict | None = None
    routing_replay: bool = False                # MoE: train with the experts the sampler routed every token to
    tree_packing: bool = False                  # store every prompt once per group; its completions attend it as branches of a tree
    push_parity_tolerance: float = 0.05         # nats; after the first push trainers and rollout copy score one fixed row (0 = off)
    rollout_prefetch: int = 0                   # rounds the rollout ranks sample ahead (0 = strictly on-policy, 1 = one update stale)
    prompts_per_round: int = 8                  # in_process rollouts: prompts sampled per round (x num_generations completions)
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    reward_terms: list[dict] | None = None      # reward composer spec for in_process rollouts on text prompts
    synthetic_reward_token: int = -1            # >= 0: tokenizer-free reward = share of completion tokens equal to it
    synthetic_reward_below: int = -1            # >= 0: tokenizer-free reward = share of completion tokens with an id below it
