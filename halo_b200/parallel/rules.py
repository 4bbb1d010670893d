"""Which parallelism layouts are accepted, and why the others are not.

Axis combinations go through an ALLOWLIST of eleven sets - anything unlisted is refused with the
mechanism that breaks it - and a listed set still has to satisfy the structural rules below
(divisibility, NVLink-domain locality, FSDP knob consistency). The pairing rules are those of the
reference (halo/distributed/parallelism_rules.py:50-67 allowlist, :380-575 structural rules);
refusals that existed only because of DeepEP's buffers (several dispatch groups racing on one
domain, the legacy-buffer topology limits) have no counterpart here because each dispatch group
owns its own peer-mapped buffers and barriers.
"""

from __future__ import annotations

from halo_b200.config_validation import ConfigError

AXES = (
    ("pp", "pipeline_parallel_size", "pp_size"),
    ("ep", "expert_parallel_size", "ep_size"),
    ("etp", "expert_tensor_parallel_size", "expert_tp_size"),
    ("tp", "tensor_parallel_size", "tp_size"),
    ("cp", "context_parallel_size", "cp_size"),
)

SUPPORTED_AXIS_SETS = frozenset(map(frozenset, (
    (), ("ep",), ("etp",), ("tp",), ("cp",), ("pp",),
    ("ep", "tp"), ("ep", "cp"), ("ep", "etp"), ("pp", "ep"), ("pp", "etp"),
)))

# the failure a refused combination would run into; a missing entry only shortens the message
MECHANISMS = {
    frozenset({"tp", "cp"}): (
        "tensor-parallel and context-parallel groups are both contiguous rank blocks, so a rank's TP partners "
        "would also be its CP partners: they would have to hold the same tokens (TP) and different sequence chunks "
        "(CP) at once, and data_parallel_size counts only the wider of the two. Use EP+TP or EP+CP."),
    frozenset({"etp", "cp"}): (
        "expert-TP partners hold slices of one expert and sum their outputs token by token, so they must see the "
        "same tokens; CP gives every rank a different chunk of the sequence. Drop one of the two."),
    frozenset({"tp", "etp"}): (
        "attention TP and expert TP would shard the same ranks along two different axes. Use EP+TP (attention "
        "sharded, experts distributed) or pure ETP."),
    frozenset({"pp", "tp"}): (
        "a pipeline stage must be made of whole NVLink domains, so PP+TP cannot start on one box, and replicated "
        "per-head norm parameters would be re-reduced on every micro-batch. Use PP+EP, or TP without PP."),
    frozenset({"pp", "cp"}): (
        "the pipeline loss is normalised per stage and carries no factor that cancels context_parallel_size, so "
        "every gradient would come out context_parallel_size times too small. Use PP or CP, not both."),
    frozenset({"pp", "ep", "etp"}): (
        "the expert-TP sum of the MoE input gradient is model math that runs inside every micro-batch backward and "
        "would interleave with the expert combine of the same backward in an order the ranks do not share. Use "
        "PP+EP or PP+ETP."),
    frozenset({"pp", "ep", "tp"}): (
        "the deferred expert-replica sweep needs the non-expert parameters sharded over the EP group while EP+TP "
        "shards them over a (dp, tp) mesh. Use PP+EP."),
    frozenset({"pp", "ep", "cp"}): (
        "under PP the expert gradients are divided by the stage width as if every rank were a data-parallel "
        "replica; CP ranks hold chunks of the same batch, so expert gradients would be context_parallel_size times "
        "too small. Use PP+EP."),
    frozenset({"ep", "tp", "etp"}): "attention TP and expert TP cannot both shard the EP group. Use EP+TP or EP+ETP.",
}


def _active(pc) -> frozenset[str]:
    return frozenset(name for name, _, attr in AXES if getattr(pc, attr) > 1)


def reject_unsupported_axes(pc) -> None:
    axes = _active(pc)
    if axes in SUPPORTED_AXIS_SETS:
        return
    named = " + ".join(f"{flag}={getattr(pc, attr)}" for name, flag, attr in AXES if name in axes)
    why = MECHANISMS.get(axes)
    if why is None:
        for bad, text in MECHANISMS.items():
            if bad <= axes:
                why = text
                break
    listed = "; ".join("+".join(sorted(s)) or "data parallel only" for s in sorted(SUPPORTED_AXIS_SETS, key=sorted))
    raise ConfigError(f"the combination {named} is not supported: {why or 'it is not on the allowlist'} "
                      f"Supported axis sets: {listed}.")


def _reject_pipeline(pc) -> None:
    if pc.pp_size == 1:
        if pc.pp_split is not None:
            raise ConfigError("pipeline_split is set but pipeline_parallel_size is 1")
        return
    if pc.stage_world_size < 2:
        raise ConfigError(
            f"pipeline_parallel_size={pc.pp_size} leaves {pc.stage_world_size} rank per stage; a stage needs at "
            f"least 2 ranks (its experts or their FFN slices are spread inside the stage)")
    if pc.stage_world_size % pc.nvlink_domain_size:
        raise ConfigError(
            f"a pipeline stage ({pc.stage_world_size} ranks) must be whole NVLink domains "
            f"({pc.nvlink_domain_size}): only the stage boundary is meant to cross domains")
    if pc.pp_split is not None:
        if len(pc.pp_split) != pc.pp_size or any((not isinstance(n, int)) or n < 1 for n in pc.pp_split):
            raise ConfigError(f"pipeline_split must list {pc.pp_size} positive layer counts, got {pc.pp_split!r}")
    if pc.pp_microbatches and pc.pp_schedule == "1f1b" and pc.pp_microbatches < pc.pp_size:
        raise ConfigError(
            f"pipeline_microbatches={pc.pp_microbatches} cannot fill a 1F1B pipeline of {pc.pp_size} stages")


def _reject_ep_group(pc) -> None:
    if pc.ep_group_size == 1:
        return
    if pc.stage_world_size % pc.ep_group_size:
        raise ConfigError(
            f"expert_parallel_size * expert_tensor_parallel_size = {pc.ep_group_size} does not divide the stage "
            f"width {pc.stage_world_size}")
    if pc.ep_scope == "node" and pc.nvlink_domain_size % pc.ep_group_size:
        raise ConfigError(
            f"a domain-local expert group of {pc.ep_group_size} ranks does not tile the NVLink domain "
            f"({pc.nvlink_domain_size}); use ep_scope='global' or a size that divides the domain")
    if pc.expert_tp_size > 1 and pc.nvlink_domain_size % pc.expert_tp_size:
        raise ConfigError(
            f"expert_tensor_parallel_size={pc.expert_tp_size} must divide the NVLink domain "
            f"({pc.nvlink_domain_size}): its token-space sums run on NVLink")
    pc.ep_layout  # noqa: B018  constructing the layout raises on a group that cannot tile the stage


def _reject_tp(pc) -> None:
    if pc.tp_size == 1:
        return
    if pc.nvlink_domain_size % pc.tp_size:
        raise ConfigError(
            f"tensor_parallel_size={pc.tp_size} must divide the NVLink domain ({pc.nvlink_domain_size}): every "
            f"layer's all-gather / reduce-scatter runs inside it")
    if pc.ep_size > 1 and pc.ep_size % pc.tp_size:
        raise ConfigError(
            f"with EP+TP, tensor_parallel_size ({pc.tp_size}) must divide expert_parallel_size ({pc.ep_size}) so a "
            f"TP group sits inside one expert group")


def _reject_cp(pc) -> None:
    if pc.cp_size == 1:
        return
    if pc.nvlink_domain_size % pc.cp_size:
        raise ConfigError(
            f"context_parallel_size={pc.cp_size} must divide the NVLink domain ({pc.nvlink_domain_size}): the K/V "
            f"ring runs over peer memory")
    if pc.ep_group_size > 1:
        if pc.ep_scope == "global":
            raise ConfigError("EP+CP needs a domain-local expert group (ep_scope='node'); a cross-domain group is "
                              "incompatible with the K/V ring")
        if pc.ep_group_size != pc.nvlink_domain_size:
            raise ConfigError(
                f"EP+CP needs the expert group to fill the NVLink domain: ep_group_size={pc.ep_group_size} "
                f"(expert_parallel_size={pc.ep_size} * expert_tensor_parallel_size={pc.expert_tp_size}) vs "
                f"nvlink_domain_size={pc.nvlink_domain_size}")


def _reject_hsdp(pc) -> None:
    if not pc.use_hsdp:
        return
    if pc.tp_size > 1 or pc.expert_tp_size > 1:
        raise ConfigError("use_hsdp is not supported with TP or expert TP: those modes build their own (dp, tp) layout")
    if pc.ep_size > 1:
        raise ConfigError("use_hsdp is not supported with EP: multi-group EP already shards over the expert group")


def _reject_fsdp_knobs(pc) -> None:
    if not pc.fsdp_reshard_after_backward and pc.fsdp_reshard_after_forward:
        raise ConfigError("fsdp_reshard_after_backward=False contradicts fsdp_reshard_after_forward=True: full "
                          "sharding exists to free parameters, keeping them gathered across the accumulation window "
                          "defeats it")
    if pc.fsdp_defer_grad_sync and pc.fsdp_reshard_after_forward:
        raise ConfigError("fsdp_defer_grad_sync=True contradicts fsdp_reshard_after_forward=True: a deferred reduce "
                          "holds every unsharded gradient across the window, the state full sharding removes")
    if not pc.fsdp_reshard_after_backward and (pc.tp_size > 1 or pc.pp_size > 1):
        raise ConfigError("fsdp_reshard_after_backward=False is only wired through the DP / CP / EP paths")
    if pc.fsdp_defer_grad_sync and (pc.pp_size > 1 or (pc.tp_size > 1 and pc.data_parallel_size == 1)):
        raise ConfigError("fsdp_defer_grad_sync=True has no per-micro-step gradient reduce to defer in this layout")
    if not pc.fsdp_shard_ep1_experts and (pc.tp_size > 1 or pc.cp_size > 1):
        raise ConfigError("fsdp_shard_ep1_experts=False is not honoured under TP or CP, which always shard the "
                          "replicated experts")
    if pc.fsdp_reshard_after_forward:
        if pc.ep_group_size > 1:
            raise ConfigError(
                f"fsdp_reshard_after_forward=True (ZeRO-3) is not supported where an expert group exists "
                f"(ep_group_size={pc.ep_group_size}): its backward all-gather would interleave with the expert "
                f"combine. Use activation checkpointing or ZeRO-2 (fsdp_reshard_after_forward=False)")
        if pc.tp_size > 1 and pc.data_parallel_size > 1:
            raise ConfigError("fsdp_reshard_after_forward=True is not supported with TP + data parallelism")


def reject_invalid_composition(pc) -> None:
    _reject_pipeline(pc)
    _reject_ep_group(pc)
    _reject_tp(pc)
    _reject_cp(pc)
    _reject_hsdp(pc)
    _reject_fsdp_knobs(pc)


# ---- model-dependent rules (need the architecture) -------------------------------------------------
def reject_model_layout(pc, model_cfg, packed: bool = True) -> None:
    """Refusals that need the model: expert / head divisibility."""
    if model_cfg.is_moe:
        if model_cfg.num_experts % pc.ep_size:
            raise ConfigError(
                f"num_experts ({model_cfg.num_experts}) is not divisible by expert_parallel_size ({pc.ep_size})")
        if pc.expert_tp_size > 1 and model_cfg.moe_intermediate_size % (pc.expert_tp_size * 8):
            raise ConfigError(
                f"moe_intermediate_size ({model_cfg.moe_intermediate_size}) must be a multiple of "
                f"8 * expert_tensor_parallel_size ({pc.expert_tp_size})")
    elif pc.ep_size > 1 or pc.expert_tp_size > 1:
        raise ConfigError("expert parallelism was requested for a model without routed experts")
    if pc.tp_size > 1:
        if model_cfg.num_attention_heads % pc.tp_size or model_cfg.num_key_value_heads % pc.tp_size:
            raise ConfigError(
                f"tensor_parallel_size ({pc.tp_size}) must divide num_attention_heads "
                f"({model_cfg.num_attention_heads}) and num_key_value_heads ({model_cfg.num_key_value_heads})")
    if getattr(model_cfg, "attention_sinks", False) or getattr(model_cfg, "expert_bias", False):
        # whole experts move between ranks (their bias rows with them), so expert parallelism is fine; nothing cuts
        # inside an expert, a head group or a row
        cut = [name for name, size in (("expert_tensor_parallel_size", pc.expert_tp_size),
                                       ("tensor_parallel_size", pc.tp_size), ("context_parallel_size", pc.cp_size)) if size > 1]
        if cut:
            raise ConfigError(f"{model_cfg.family}: attention sinks and experts with bias vectors are not cut inside an expert, "
                              f"a head group or a row (data, expert and pipeline parallelism only); drop {', '.join(cut)}")
    masked_only = [what for what, on in (("a sliding window", getattr(model_cfg, "sliding_window", 0)),
                                         ("a configured softmax scale", (getattr(model_cfg, "query_pre_attn_scalar", 0) or model_cfg.head_dim) != model_cfg.head_dim),
                                         ("a tanh-GELU gate", getattr(model_cfg, "hidden_activation", "silu") != "silu")) if on]
    if masked_only and (pc.tp_size > 1 or pc.cp_size > 1):
        raise ConfigError(f"{model_cfg.family}: {', '.join(masked_only)} run on whole rows with all heads on every rank; drop "
                          f"tensor_parallel_size / context_parallel_size")
    if getattr(model_cfg, "kv_lora_rank", 0) and (pc.tp_size > 1 or pc.cp_size > 1):
        raise ConfigError(f"{model_cfg.family}: latent attention runs on whole rows with all heads on every rank; drop "
                          f"tensor_parallel_size / context_parallel_size (expert and pipeline parallelism are fine)")
    if getattr(model_cfg, "conv_kernel", 0) and (pc.tp_size > 1 or pc.cp_size > 1):
        raise ConfigError(f"{model_cfg.family}: the short-convolution mixer reads a token's predecessors in its row, so rows are not "
                          f"cut; drop tensor_parallel_size / context_parallel_size (expert and pipeline parallelism are fine)")
    if (getattr(model_cfg, "linear_num_value_heads", 0) or getattr(model_cfg, "attn_output_gate", False)) and (pc.tp_size > 1 or pc.cp_size > 1):
        raise ConfigError(f"{model_cfg.family}: the gated delta-rule layers carry a state along the row and the gated attention keeps "
                          f"all heads on every rank, so rows and heads are not cut; drop tensor_parallel_size / context_parallel_size "
                          f"(expert and pipeline parallelism are fine)")
    if pc.pp_size > 1 and model_cfg.num_hidden_layers < pc.pp_size:
        raise ConfigError(f"{model_cfg.num_hidden_layers} layers cannot fill {pc.pp_size} pipeline stages")
