"""GRPO entry point. Where a round's rollouts come from:

* ``rollout_gpus: N`` with a reward configured - the last ``N`` ranks hold a serving copy of the policy, receive the
  weights after every optimizer step, sample the trainers' rounds from it and publish them through the rendezvous
  store (``rollout_prefetch`` rounds ahead);
* ``rollout_backend: in_process`` - the trainer's own weights sample every round;
* ``environment_type`` - either of the above plays environment episodes (multi-turn, tools) instead of single turns;
* ``dataset_path`` of scored generations - offline GRPO; nothing - synthetic rollouts of the benchmark's shape.

With ``grpo_beta > 0`` a frozen copy of the starting policy anchors the KL term."""

import json

import numpy as np

from halo_b200.configs.arguments import GRPOArguments
from halo_b200.entrypoints.script import (build_runtime, init_training_script, load_policy_model, parse_script_args,
                                          run_trainer, with_distributed_teardown)


def rollouts_from_jsonl(path: str, group: int, dp_rank: int = 0, dp_size: int = 1, seed: int = 0, epochs: float = 1.0,
                        prompts_per_round: int = 64, shuffle: bool = True):
    """Each line: {"prompt_ids": [...], "completion_ids": [...], "reward": x, "sampler_logps": [...]?, "group_id": g?}.
    Without ``group_id`` every ``group`` consecutive lines are one prompt's generations. A data-parallel rank trains on
    its own contiguous cut of the groups, ``prompts_per_round`` groups per round, reshuffled every epoch with a seed all
    ranks share (:class:`halo_b200.trainers.grpo.group_sampler.GroupSampler`)."""
    from halo_b200.trainers.grpo.group_sampler import GroupSampler
    from halo_b200.trainers.grpo.trainer import Rollout

    rows = [json.loads(l) for l in open(path) if l.strip()]
    ids = [r["group_id"] if "group_id" in r else i // group for i, r in enumerate(rows)]
    sampler = GroupSampler(ids, dp_rank, dp_size, prompts_per_round, shuffle, seed)

    def source(round_index: int):
        picked = sampler.round_rows(round_index, epochs)
        if picked is None:
            return None
        return [Rollout(np.asarray(r["prompt_ids"]), np.asarray(r["completion_ids"]),
                        None if r.get("sampler_logps") is None else np.asarray(r["sampler_logps"], dtype=np.float32),
                        float(r["reward"])) for r in (rows[i] for i in picked)]

    source.sampler = sampler
    return source


def has_live_reward(grpo_args) -> bool:
    return (grpo_args.synthetic_reward_token >= 0 or grpo_args.synthetic_reward_below >= 0 or bool(grpo_args.reward_terms)
            or bool(grpo_args.environment_type))


def in_process_source(model, model_args, data_args, train_args, grpo_args, pc):
    """On-policy rollouts sampled from the trainer's own weights (``rollout_backend: in_process``)."""
    return sampling_source(model, model_args, data_args, train_args, grpo_args, pc.data_parallel_rank, pc.data_parallel_size)


def prompts_and_reward(vocab_size: int, model_args, data_args, train_args, grpo_args, consumer_rank: int, n_consumers: int):
    """``(prompts, reward_fn, tokenizer or None)`` of single-turn sampled rollouts for one consumer."""
    from halo_b200.trainers.grpo.online import text_reward, token_below_reward, token_match_reward

    tokenizer = None
    if data_args.dataset_path:
        rows = [json.loads(l) for l in open(data_args.dataset_path) if l.strip()]
        rows = rows[consumer_rank::max(1, n_consumers)]
        if rows and "prompt_ids" not in rows[0]:
            from halo_b200.entrypoints.script import load_tokenizer

            tokenizer = load_tokenizer(model_args)
            for r in rows:
                r["prompt_ids"] = tokenizer(r["prompt"])["input_ids"]
        prompts = rows
    else:
        rng = np.random.default_rng(train_args.seed + consumer_rank)
        vocab = data_args.synthetic_vocab or vocab_size
        prompts = [rng.integers(0, vocab, size=int(rng.integers(4, min(32, grpo_args.max_prompt_length) + 1))) for _ in range(256)]
    if grpo_args.synthetic_reward_token >= 0:
        reward = token_match_reward(grpo_args.synthetic_reward_token)
    elif grpo_args.synthetic_reward_below >= 0:
        reward = token_below_reward(grpo_args.synthetic_reward_below)
    elif grpo_args.reward_terms:
        from halo_b200.entrypoints.script import load_tokenizer
        from halo_b200.rewards.terms import RewardComposer, parse_terms

        tokenizer = tokenizer or load_tokenizer(model_args)
        reward = text_reward(tokenizer, RewardComposer(parse_terms(grpo_args.reward_terms)))
    else:
        raise ValueError("sampled rollouts need reward_terms (text prompts) or synthetic_reward_token")
    return prompts, reward, tokenizer


def sampling_source(model, model_args, data_args, train_args, grpo_args, consumer_rank: int, n_consumers: int):
    """A source that samples from ``model`` for consumer ``consumer_rank`` of ``n_consumers``. Prompts: a JSONL of
    {"prompt_ids": [...]} or {"prompt": "..."} rows (each consumer takes its stride), else random ones."""
    from halo_b200.inference.generate import SamplingParams
    from halo_b200.trainers.grpo.online import OnPolicyRolloutSource

    if grpo_args.environment_type:
        from halo_b200.entrypoints.script import load_tokenizer
        from halo_b200.trainers.grpo.environment_rollouts import EnvironmentRolloutSource

        if not data_args.dataset_path:
            raise ValueError("environment rollouts need dataset_path: a JSONL of task rows for the environment")
        tasks = [json.loads(l) for l in open(data_args.dataset_path) if l.strip()][consumer_rank::max(1, n_consumers)]
        composer = None
        if grpo_args.reward_terms:
            from halo_b200.rewards.terms import RewardComposer, parse_terms

            composer = RewardComposer(parse_terms(grpo_args.reward_terms))
        sampling = SamplingParams(max_new_tokens=grpo_args.max_completion_length, temperature=grpo_args.temperature,
                                  top_k=grpo_args.top_k, top_p=grpo_args.top_p)
        return EnvironmentRolloutSource(model, load_tokenizer(model_args), tasks, grpo_args.environment_type, grpo_args.num_generations,
                                        sampling, grpo_args.prompts_per_round, composer, grpo_args.environment_options,
                                        seed=train_args.seed + consumer_rank)
    prompts, reward, tokenizer = prompts_and_reward(model.cfg.vocab_size, model_args, data_args, train_args, grpo_args,
                                                    consumer_rank, n_consumers)
    eos = getattr(tokenizer, "eos_token_id", None) if tokenizer is not None else None
    sampling = SamplingParams(max_new_tokens=grpo_args.max_completion_length, temperature=grpo_args.temperature,
                              top_k=grpo_args.top_k, top_p=grpo_args.top_p)
    return OnPolicyRolloutSource(model, prompts, reward, grpo_args.num_generations, sampling, grpo_args.prompts_per_round,
                                 eos_token_id=eos, seed=train_args.seed + consumer_rank,
                                 max_prompt_length=grpo_args.max_prompt_length, record_routing=grpo_args.routing_replay)


def server_source(model, model_args, data_args, train_args, grpo_args, pc, device):
    """Rollouts from a generation server outside the job (``rollout_backend: vllm`` / ``sglang``): every trainer samples
    its own prompts' completions over HTTP; global rank 0 also holds the weight-sync client. The server is checked before
    the first round (reachable, long enough context, returns sampled token ids, takes a weight update)."""
    from halo_b200.trainers.grpo.engine_preflight import run_preflight
    from halo_b200.weight_sync.clients import make_client
    from halo_b200.weight_sync.engine_push import ServerRolloutSource

    if not grpo_args.rollout_server_url:
        raise ValueError(f"rollout_backend: {grpo_args.rollout_backend} needs rollout_server_url (http://host:port of the server)")
    if grpo_args.environment_type:
        raise ValueError("environment episodes are played against a policy inside the job (rollout_gpus or in_process), "
                         "not against an external server")
    prompts, reward, _ = prompts_and_reward(model.cfg.vocab_size, model_args, data_args, train_args, grpo_args,
                                            pc.data_parallel_rank, pc.data_parallel_size)
    model_id = grpo_args.rollout_served_model or model_args.model_name_or_path
    client = None
    if pc.global_rank == 0:
        client = make_client(grpo_args.rollout_backend, grpo_args.rollout_server_url, model_id=model_id,
                             chunk_bytes=grpo_args.weight_sync_chunk_mb << 20)
        run_preflight(client, model.cfg, grpo_args)
    source = ServerRolloutSource(grpo_args.rollout_server_url, model_id, prompts, reward, grpo_args.num_generations,
                                 grpo_args.max_completion_length, grpo_args.temperature, grpo_args.top_p, grpo_args.top_k,
                                 grpo_args.prompts_per_round, grpo_args.max_prompt_length)
    return source, client


def serve_rollout_copy(model_args, pc, device, roles, grpo_args, data_args=None, train_args=None):
    """A rollout rank: hold a full (unsharded) serving copy and take every pushed update; with a reward configured
    it also samples the trainers' rounds from that copy and publishes them through the rendezvous store."""
    import torch

    from halo_b200.models.config import PRESETS, ModelConfig
    from halo_b200.models.qwen3 import build_model
    from halo_b200.weight_sync.group import build_manifest
    from halo_b200.weight_sync.roles import make_sync, rollout_loop

    cfg = PRESETS[model_args.model_preset]() if model_args.init_from_scratch else ModelConfig.load(model_args.model_name_or_path)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    if model_args.init_from_scratch:
        serving = build_model(cfg, device=device, dtype=dtype, transport=None, gradient_checkpointing=False)
    else:
        # the first rounds are sampled before any push arrives: the copy starts from the same checkpoint as the trainers
        from halo_b200.checkpoint.load import from_pretrained

        serving = from_pretrained(model_args.model_name_or_path, device=device, dtype=dtype, gradient_checkpointing=False)
    sync = make_sync(roles, device, build_manifest(serving), grpo_args.weight_sync_chunk_mb << 20)
    publisher = None
    if has_live_reward(grpo_args):
        import torch.distributed as dist

        from halo_b200.trainers.grpo.remote_rollouts import RolloutPublisher, served_trainers

        mine = served_trainers(roles.rollout_ranks.index(roles.rank), len(roles.rollout_ranks), len(roles.trainer_ranks))
        publisher = RolloutPublisher(
            dist.distributed_c10d._get_default_store(), mine,
            lambda t: sampling_source(serving, model_args, data_args, train_args, grpo_args, t, len(roles.trainer_ranks)),
            prefetch=grpo_args.rollout_prefetch)
        publisher.start()
    first_rollout_rank = roles.rank == roles.rollout_ranks[0]

    def on_update(n_updates: int) -> None:
        if n_updates == 1 and first_rollout_rank and grpo_args.push_parity_tolerance > 0:
            import torch.distributed as dist

            from halo_b200.weight_sync import parity

            parity.publish(dist.distributed_c10d._get_default_store(), parity.score_fixed_row(serving, device))
        if publisher is not None:
            publisher.on_update(n_updates)

    n = rollout_loop(sync, roles, device, dict(serving.named_parameters()), on_update=on_update)
    return {"updates": n, "rounds": publisher.next_round if publisher is not None else 0}


@with_distributed_teardown
def main(argv=None):
    from halo_b200.trainers.grpo.trainer import GRPOTrainer, synthetic_rollouts

    device, (model_args, data_args, train_args, par_args, grpo_args) = parse_script_args(GRPOArguments, argv=argv)
    roles = None
    if grpo_args.rollout_gpus > 0 and getattr(model_args, "use_peft", False):
        raise ValueError("rollout_gpus with use_peft: pushing adapters to the rollout copy is not built; sample in process "
                         "(rollout_backend: in_process) or train full weights")
    if grpo_args.rollout_gpus > 0:
        from halo_b200.weight_sync.roles import split_roles

        roles = split_roles(grpo_args.rollout_gpus)
    pc = init_training_script(device, model_args, train_args, par_args,
                              world_size=len(roles.trainer_ranks) if roles else 0,
                              global_rank=(roles.rank if roles.is_trainer else 0) if roles else -1)
    if roles is not None and not roles.is_trainer:
        return serve_rollout_copy(model_args, pc, device, roles, grpo_args, data_args, train_args)
    runtime = build_runtime(pc, device, group=roles.trainer_group if roles else None)
    model = load_policy_model(model_args, pc, device, runtime, train_args.gradient_checkpointing,
                              max_tokens=grpo_args.token_budget)
    runtime = getattr(model, "parallel_runtime", runtime)      # tensor / context parallelism finish their runtime there
    engine_client = None
    if roles is not None and has_live_reward(grpo_args):
        import torch.distributed as dist

        from halo_b200.trainers.grpo.remote_rollouts import StoreRolloutSource

        source = StoreRolloutSource(dist.distributed_c10d._get_default_store(), roles.rank)     # sampled on the rollout ranks
    elif grpo_args.rollout_backend in ("vllm", "sglang"):
        source, engine_client = server_source(model, model_args, data_args, train_args, grpo_args, pc, device)
    elif grpo_args.rollout_backend == "in_process":
        source = in_process_source(model, model_args, data_args, train_args, grpo_args, pc)
    elif data_args.dataset_path:
        source = rollouts_from_jsonl(data_args.dataset_path, grpo_args.num_generations, pc.data_parallel_rank,
                                     pc.data_parallel_size, seed=train_args.seed, epochs=train_args.num_train_epochs)
    else:
        vocab = data_args.synthetic_vocab or model.cfg.vocab_size

        def source(i):
            return synthetic_rollouts(i, n_prompts=8, n_generations=grpo_args.num_generations, vocab=vocab,
                                      prompt_len=(8, min(64, grpo_args.max_prompt_length)),
                                      response_len=(8, min(256, grpo_args.max_completion_length)),
                                      seed=train_args.seed + pc.data_parallel_rank)
    weight_sync = None
    if engine_client is not None or (grpo_args.rollout_backend in ("vllm", "sglang") and getattr(model_args, "use_peft", False)):
        if getattr(model_args, "use_peft", False) and not getattr(model_args, "merge_adapters_on_save", False):
            # adapters travel as files the server loads under a versioned name; rollouts ask for that name
            import os

            from halo_b200.weight_sync.adapter_push import AdapterPusher

            weight_sync = AdapterPusher(engine_client, os.path.join(train_args.output_dir, "served_adapters"))
            source.model_id = weight_sync.current_model_id or source.model_id
            pusher, plain_push = weight_sync, weight_sync.push

            def push_and_rename(m):
                plain_push(m)
                source.model_id = pusher.current_model_id

            weight_sync.push = push_and_rename
        else:
            from halo_b200.weight_sync.engine_push import EngineWeightPusher

            weight_sync = EngineWeightPusher(engine_client, device, runtime.ep_group if runtime else None)
    if roles is not None:
        from halo_b200.weight_sync.group import full_manifest
        from halo_b200.weight_sync.roles import ModelWeightPusher, make_sync

        sync = make_sync(roles, device, full_manifest(model), grpo_args.weight_sync_chunk_mb << 20)
        weight_sync = ModelWeightPusher(sync, roles, device, runtime.ep_group if runtime else None)
        if grpo_args.push_parity_tolerance > 0:
            weight_sync.parity_tolerance = grpo_args.push_parity_tolerance
    ref_model = None
    if grpo_args.grpo_beta > 0:
        # the KL anchor: a frozen copy of the policy as it starts (same weights, same sharding, never updated)
        import copy

        import torch

        base_args = copy.copy(model_args)
        if getattr(base_args, "use_peft", False):
            base_args.use_peft, base_args.adapter_path, base_args.merge_adapters_on_save = False, "", False
        ref_model = load_policy_model(base_args, pc, device, runtime, False, max_tokens=grpo_args.token_budget)
        for p in ref_model.parameters():
            p.requires_grad_(False)
        ref_model.eval()
        torch.manual_seed(train_args.seed)
    if grpo_args.sdpg_beta_base > 0:
        from halo_b200.entrypoints.script import load_tokenizer
        from halo_b200.trainers.grpo.sdpg import HintedSource, SDPGTrainer

        if roles is not None and has_live_reward(grpo_args):
            raise ValueError("sdpg_beta_base > 0 needs each rollout's task row on the trainer; rounds published by rollout "
                             "ranks carry tokens only (use rollout_backend: in_process, vllm or sglang)")
        if not data_args.dataset_path:
            raise ValueError("sdpg_beta_base > 0 needs dataset_path: task rows with a prompt and the gold answer the hint reveals")
        source = HintedSource(source, load_tokenizer(model_args), grpo_args.sdpg_answer_field, grpo_args.sdpg_hint_template)
        trainer = SDPGTrainer(model, train_args, source, grpo_args=grpo_args, ref_model=ref_model, weight_sync=weight_sync,
                              device=device, parallel=runtime, parallelism_fingerprint=pc.fingerprint(),
                              sdpg_beta_base=grpo_args.sdpg_beta_base, sdpg_beta_warmup_steps=grpo_args.sdpg_beta_warmup_steps,
                              sdpg_beta_decay_steps=grpo_args.sdpg_beta_decay_steps, sdpg_loss=grpo_args.sdpg_loss,
                              sdpg_temperature=grpo_args.sdpg_temperature,
                              opd_positive_advantage_only=grpo_args.opd_positive_advantage_only)
    else:
        trainer = GRPOTrainer(model, train_args, source, grpo_args=grpo_args, ref_model=ref_model, weight_sync=weight_sync,
                              device=device, parallel=runtime, parallelism_fingerprint=pc.fingerprint())
    if roles is not None:
        trainer.collective_group = roles.trainer_group       # the rollout ranks take no part in saves and barriers
        trainer.rank = roles.rank
    try:
        return run_trainer(trainer, train_args)
    finally:
        if weight_sync is not None:
            weight_sync.close()


if __name__ == "__main__":
    main()
