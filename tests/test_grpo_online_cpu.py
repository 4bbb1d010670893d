"""On-policy GRPO end to end on CPU: the policy samples its own rollouts, a verifiable reward scores them, and
training raises the mean reward; the sampler's log-probabilities line up with the trainer's."""

import numpy as np
import pytest
import torch

from halo_b200.configs.arguments import GRPOArguments, TrainingArguments
from halo_b200.inference.generate import SamplingParams
from halo_b200.models.config import ModelConfig
from halo_b200.models.qwen3 import build_model
from halo_b200.trainers.grpo.online import OnPolicyRolloutSource, token_match_reward
from halo_b200.trainers.grpo.trainer import GRPOTrainer, build_grpo_batch


def tiny():
    return ModelConfig(vocab_size=32, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                       head_dim=16, intermediate_size=64, moe_intermediate_size=0, num_experts=0, model_type="qwen3")


def test_sampler_logprobs_are_the_trainers(tmp_path):
    model = build_model(tiny(), device="cpu", seed=0, gradient_checkpointing=False)
    prompts = [np.array([1, 2, 3, 4]), np.array([5, 6])]
    src = OnPolicyRolloutSource(model, prompts, token_match_reward(7), num_generations=2, sampling=SamplingParams(max_new_tokens=5),
                                prompts_per_round=2, seed=1)
    rollouts = src(0)
    assert len(rollouts) == 4 and all(len(r.completion_ids) == 5 for r in rollouts)
    batch = build_grpo_batch(rollouts, torch.zeros(4), torch.zeros(4, dtype=torch.bool))
    with torch.no_grad():
        logp, _ = model.token_logprobs(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
    scored = batch.old_logprobs != 0
    assert int(scored.sum()) == 20
    assert torch.allclose(logp[scored], batch.old_logprobs[scored], atol=1e-4)


@pytest.mark.parametrize("tree", [False, True])
def test_on_policy_grpo_raises_the_reward(tmp_path, tree):
    torch.manual_seed(0)
    model = build_model(tiny(), device="cpu", seed=0, gradient_checkpointing=False)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 32, size=int(rng.integers(3, 8))) for _ in range(16)]
    src = OnPolicyRolloutSource(model, prompts, token_match_reward(7), num_generations=8,
                                sampling=SamplingParams(max_new_tokens=8), prompts_per_round=4, seed=3, rounds=40)
    args = TrainingArguments(output_dir=str(tmp_path / "run"), max_steps=40, learning_rate=2e-2, optim="adamw_torch",
                             lr_scheduler_type="constant", weight_decay=0.0, logging_steps=1000, gradient_checkpointing=False)
    trainer = GRPOTrainer(model, args, src, device=torch.device("cpu"),
                          grpo_args=GRPOArguments(num_generations=8, max_completion_length=8, token_budget=4096, tree_packing=tree))
    rewards = []
    trainer.callbacks.append(type("Track", (), {"on_step_end": lambda self, t, logs=None: rewards.append(src.mean_reward),
                                                "__getattr__": lambda self, name: (lambda *a, **k: None)})())
    trainer.train()
    assert np.mean(rewards[:5]) < 0.15                   # a fresh policy emits token 7 about once in 32
    assert np.mean(rewards[-5:]) > np.mean(rewards[:5]) + 0.3, (rewards[:5], rewards[-5:])


def test_split_job_samples_on_the_rollout_rank(tmp_path):
    """One trainer rank and one rollout rank (gloo): the rollout rank samples every round from its serving copy,
    which follows the trainer's weights, and the reward rises."""
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "grpo.yaml"
    cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\nmax_steps: 12\noptim: adamw_torch\nlearning_rate: 2.0e-2\n"
                   "lr_scheduler_type: constant\nweight_decay: 0.0\n"
                   f"output_dir: {tmp_path}/run\nnum_generations: 8\nprompts_per_round: 4\ntoken_budget: 4096\n"
                   "max_completion_length: 8\nmax_prompt_length: 16\nrollout_gpus: 1\nsynthetic_reward_below: 2048\nsynthetic_vocab: 64\n"
                   "rollout_prefetch: 1\n")
    r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "grpo", str(cfg), "-n", "2", "--port", "29697"],
                       cwd=root, capture_output=True, text=True, timeout=420, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    rewards = [float(x) for x in re.findall(r"rollout_reward ([0-9.]+)", out)]
    assert len(rewards) >= 10, out[-2000:]
    assert 0.3 < rewards[0] < 0.7 and max(rewards[-3:]) > rewards[0] + 0.1, rewards


def test_trust_region_breaker_skips_the_update(tmp_path):
    """Rollouts whose sampler log-probabilities are far from the trainer's put every token at the importance cap:
    with the breaker armed the weights stay put, without it they move."""
    from halo_b200.trainers.grpo.trainer import Rollout

    def run(fraction):
        model = build_model(tiny(), device="cpu", seed=0, gradient_checkpointing=False)
        before = {n: p.detach().clone() for n, p in model.named_parameters()}
        rng = np.random.default_rng(1)

        def source(i):
            if i >= 2:
                return None
            out = []
            for _ in range(2):
                prompt = rng.integers(0, 32, size=4)
                for _ in range(4):
                    comp = rng.integers(0, 32, size=6)
                    out.append(Rollout(prompt, comp, np.full(6, -30.0, dtype=np.float32), float(rng.normal())))
            return out

        args = TrainingArguments(output_dir=str(tmp_path / f"r{fraction}"), max_steps=2, learning_rate=1e-2, optim="adamw_torch",
                                 weight_decay=0.0, lr_scheduler_type="constant", logging_steps=1000)
        trainer = GRPOTrainer(model, args, source, device=torch.device("cpu"),
                              grpo_args=GRPOArguments(num_generations=4, max_completion_length=6, token_budget=4096,
                                                      trust_region_mask_fraction=fraction))
        trainer.train()
        return max(float((p.detach() - before[n]).abs().max()) for n, p in model.named_parameters())

    assert run(0.5) == 0.0
    assert run(1.0) > 0.0


def test_tree_packing_gives_the_flat_loss_and_gradients(tmp_path):
    """The same round, flat (every completion carries its prompt) and tree-packed (each prompt stored once): the
    objective, its gradients and the per-token log-probabilities agree; the tree row is shorter."""
    from halo_b200.trainers.grpo import advantages as adv_mod
    from halo_b200.trainers.grpo.trainer import Rollout, build_grpo_tree_batch

    rng = np.random.default_rng(5)
    G, rollouts = 3, []
    for plen in (9, 5):
        prompt = rng.integers(0, 32, size=plen)
        for _ in range(G):
            n = int(rng.integers(3, 8))
            mask = np.ones(n, dtype=np.int64)
            mask[rng.integers(0, n)] = 0                                       # an environment token inside the completion
            rollouts.append(Rollout(prompt, rng.integers(0, 32, size=n), -rng.random(n).astype(np.float32), float(rng.normal()), mask))
    rewards = torch.tensor([r.reward for r in rollouts])
    adv, deg = adv_mod.group_advantages(rewards, G, "group", 0.0)
    flat = build_grpo_batch(rollouts, adv, deg)
    tree = build_grpo_tree_batch(rollouts, adv, deg, G)
    assert tree.input_ids.numel() == flat.input_ids.numel() - (G - 1) * (8 + 4)
    assert int((tree.labels != -100).sum()) == int((flat.labels != -100).sum())

    def run(batch):
        model = build_model(tiny(), device="cpu", seed=0, gradient_checkpointing=False)
        args = TrainingArguments(output_dir=str(tmp_path / "x"), max_steps=1, optim="adamw_torch", logging_steps=1000)
        trainer = GRPOTrainer(model, args, lambda i: None, device=torch.device("cpu"),
                              grpo_args=GRPOArguments(num_generations=G, max_completion_length=8, num_iterations=2))
        trainer._round_tokens = 1.0
        loss = trainer.compute_loss(model, batch, None)
        loss.backward()
        return loss.item(), {n: p.grad.clone() for n, p in model.named_parameters()}

    loss_flat, g_flat = run(flat)
    loss_tree, g_tree = run(tree)
    assert abs(loss_flat - loss_tree) < 1e-5 and abs(loss_flat) > 1e-3
    for n in g_flat:
        assert torch.allclose(g_flat[n], g_tree[n], atol=1e-5, rtol=1e-3), n


def test_routing_replay_trains_with_the_samplers_experts(tmp_path):
    """The sampler records the experts of every token it processed; a trainer whose router has drifted still routes
    those tokens as the sampler did (and routes the one unseen token of each row itself)."""
    import dataclasses

    from halo_b200.models.config import tiny_moe_config

    cfg = dataclasses.replace(tiny_moe_config(), num_hidden_layers=2, vocab_size=64)
    sampler = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
    prompts = [np.array([1, 2, 3, 4, 5]), np.array([6, 7, 8])]
    src = OnPolicyRolloutSource(sampler, prompts, token_match_reward(7), num_generations=2, sampling=SamplingParams(max_new_tokens=4),
                                prompts_per_round=2, seed=1, record_routing=True)
    rollouts = src(0)
    r = rollouts[0]
    assert r.routing.shape == (2, len(r.prompt_ids) + len(r.completion_ids) - 1, cfg.num_experts_per_tok) and r.routing_layers == [0, 1]
    batch = build_grpo_batch(rollouts, torch.zeros(4), torch.zeros(4, dtype=torch.bool))
    assert set(batch.replay_routing) == {0, 1} and int((batch.replay_routing[0] < 0).all(-1).sum()) == 4     # one unseen token per row
    # the sampler's own forward over the packed rows picks the same experts as it did while sampling
    records = []
    ctx = sampler.make_context(batch.position_ids.reshape(-1), batch.cu_seqlens, record_routing=records)
    with torch.no_grad():
        sampler.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens, ctx)
    for li in (0, 1):
        known = (batch.replay_routing[li] >= 0).all(-1)
        assert torch.equal(records[li][1][known].sort(-1).values, batch.replay_routing[li][known].sort(-1).values)
    # a trainer with a different router: free routing differs, replayed routing is the sampler's
    trainer_model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=True)
    with torch.no_grad():
        for layer in trainer_model.layers:
            layer.mlp.gate.copy_(torch.randn(layer.mlp.gate.shape, generator=torch.Generator().manual_seed(5)))
    free, forced = [], []
    with torch.no_grad():
        trainer_model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens,
                                    trainer_model.make_context(batch.position_ids.reshape(-1), batch.cu_seqlens, record_routing=free))
        trainer_model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens,
                                    trainer_model.make_context(batch.position_ids.reshape(-1), batch.cu_seqlens, record_routing=forced,
                                                               replay_topk=batch.replay_routing))
    known = (batch.replay_routing[0] >= 0).all(-1)
    assert not torch.equal(free[0][1][known], batch.replay_routing[0][known])
    assert torch.equal(forced[0][1][known], batch.replay_routing[0][known])
    assert torch.equal(forced[0][1][~known], free[0][1][~known])                       # unseen tokens route for themselves
    # and a training step with replay (under recomputation, which runs every layer twice) goes through
    args = TrainingArguments(output_dir=str(tmp_path / "run"), max_steps=1, optim="adamw_torch", logging_steps=1000)
    t = GRPOTrainer(trainer_model, args, lambda i: rollouts if i == 0 else None, device=torch.device("cpu"),
                    grpo_args=GRPOArguments(num_generations=2, max_completion_length=4, routing_replay=True))
    t.train()
    assert t.global_step == 1
