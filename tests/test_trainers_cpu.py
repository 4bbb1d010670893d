"""Objectives and trainer spine on CPU: closed-form checks of the losses, GRPO pieces, micro-batch
planning, and save / resume of a short SFT run."""

import math
import os

import numpy as np
import pytest
import torch

from halo_b200.configs.arguments import GRPOArguments, PreferenceArguments, TrainingArguments
from halo_b200.data.packing import pack_documents, synthetic_packed_batch
from halo_b200.models.config import ModelConfig
from halo_b200.models.qwen3 import build_model
from halo_b200.trainers import losses
from halo_b200.trainers.base import Trainer, newest_complete_checkpoint
from halo_b200.trainers.grpo import advantages, microbatch, objective
from halo_b200.trainers.grpo.trainer import GRPOTrainer, synthetic_rollouts
from halo_b200.trainers.preference import PreferenceBatch, PreferenceTrainer


def _tiny(seed=0, moe=False):
    cfg = ModelConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                      head_dim=32, intermediate_size=128, moe_intermediate_size=32, num_experts=4 if moe else 0,
                      num_experts_per_tok=2, model_type="qwen3_moe" if moe else "qwen3")
    return cfg, build_model(cfg, device="cpu", seed=seed)


def test_dpo_matches_closed_form_and_kto_sign():
    pc, pr, rc, rr = (torch.tensor([x]) for x in (-10.0, -12.0, -11.0, -11.5))
    loss, cw, rw = losses.dpo_loss(pc, pr, rc, rr, beta=0.5)
    assert abs(loss.item() - (-math.log(1 / (1 + math.exp(-0.5 * 1.5))))) < 1e-6
    assert cw.item() == pytest.approx(0.5) and rw.item() == pytest.approx(-0.25)
    good = losses.kto_loss(torch.tensor([0.0]), torch.tensor([-1.0]), torch.tensor([True]), torch.tensor(0.0))
    bad = losses.kto_loss(torch.tensor([0.0]), torch.tensor([-1.0]), torch.tensor([False]), torch.tensor(0.0))
    assert good.item() < 0.5 < bad.item()


def test_segment_sums_and_divergences():
    v = torch.arange(6.0)
    assert losses.segment_sums(v, [0, 2, 6]).tolist() == [1.0, 14.0]
    a = torch.randn(5, 11)
    assert losses.distillation_divergence(a, a).abs().item() < 1e-6
    assert losses.distillation_divergence(a, torch.randn(5, 11), "jsd").item() > 0


def test_group_advantages_and_degenerate_groups():
    r = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 5.0, 5.0, 5.0])
    adv, deg = advantages.group_advantages(r, 4, "group")
    assert adv[:4].sum().abs().item() < 1e-5 and adv[4:].abs().max().item() == 0
    assert deg.tolist() == [False] * 4 + [True] * 4
    adv_none, _ = advantages.group_advantages(r, 4, "none")
    assert adv_none[:4].tolist() == [-1.5, -0.5, 0.5, 1.5]
    with pytest.raises(ValueError):
        advantages.group_advantages(torch.tensor([float("nan"), 1.0]), 2)
    assert advantages.offline_group_advantages(r, 4, "minmax")[:4].tolist() == pytest.approx([-1, -1 / 3, 1 / 3, 1], abs=1e-3)


def test_clipped_objective_and_importance_weights():
    logp = torch.tensor([0.0, 0.0, 0.0], requires_grad=True)
    old = torch.tensor([0.0, -1.0, 1.0])
    adv = torch.tensor([1.0, 1.0, -1.0])
    num, per = objective.grpo_token_loss(logp, old, adv, torch.ones(3, dtype=torch.bool), 0.2, 0.28)
    assert per[0].item() == pytest.approx(-1.0)
    assert per[1].item() == pytest.approx(-1.28)            # ratio e > 1.28: clipped for a positive advantage
    assert per[2].item() == pytest.approx(0.8)              # ratio 1/e < 0.8: clipped for a negative one
    num.backward()
    assert logp.grad[1].item() == 0 and logp.grad[2].item() == 0 and logp.grad[0].item() == pytest.approx(-1.0)
    w = objective.importance_weights(torch.tensor([-1.0, 1.0, 3.0]), torch.tensor([-1.0, -1.0, 0.0]),
                                     torch.tensor([True, True, True]), 2.0)
    assert w.tolist() == [1.0, 2.0, 1.0]                    # on-policy, capped, and a token the sampler was certain of
    assert objective.k3_kl(torch.tensor([0.0]), torch.tensor([100.0])).item() == pytest.approx(math.exp(5) - 6)
    # a capped token keeps a restoring gradient: the ceiling comes from the detached policy value
    lp = torch.tensor([-9.0, -1.0], requires_grad=True)
    objective.k3_kl(lp, torch.tensor([0.0, -1.2])).sum().backward()
    assert lp.grad[0].item() == pytest.approx(1.0 - math.exp(5), rel=1e-5)     # d/dlogp (exp(d) - d - 1) at d = 5
    assert lp.grad[1].item() == pytest.approx(1.0 - math.exp(-0.2), rel=1e-5) and lp.grad[0].item() < -100


def test_round_denominators_by_loss_type():
    counted, deg = [10, 0, 6, 4], [False, False, True, False]
    assert objective.round_denominator("dapo", counted, deg, 32) == 14.0
    assert objective.round_denominator("bnpo", counted, deg, 32) == 14.0
    assert objective.round_denominator("dr_grpo", counted, deg, 32) == 128.0
    assert objective.round_denominator("grpo", counted, deg, 32) == 3.0
    with pytest.raises(ValueError):
        objective.round_denominator("other", counted, deg, 32)


def test_microbatch_plan_is_world_uniform():
    lens = [900, 800, 300, 200, 100, 50]
    bins = microbatch.first_fit_decreasing(lens, 1000)
    assert all(sum(lens[i] for i in b) <= 1000 for b in bins) and sorted(i for b in bins for i in b) == list(range(6))
    padded = microbatch.plan_microbatches([100], 1000, world_max_bins=lambda n: 3)
    assert [len(b) for b in padded] == [0, 0, 1]            # idle slots lead, the real backward is last
    dealt = microbatch.deal_rows_across_ranks(lens, 2)
    assert sorted(len(d) for d in dealt) == [3, 3]
    with pytest.raises(ValueError):
        microbatch.first_fit_decreasing([2000], 1000)


def test_sft_save_resume_is_exact(tmp_path):
    cfg, _ = _tiny()
    batches = [synthetic_packed_batch(128, cfg.vocab_size, seed=i, lo=16, hi=64) for i in range(8)]

    def run(steps, out, resume=""):
        _, model = _tiny()
        args = TrainingArguments(output_dir=str(out), max_steps=6, learning_rate=1e-2, save_steps=3,
                                 optim="adamw_torch", lr_scheduler_type="linear", logging_steps=1)
        t = Trainer(model, args, batches[:steps], device="cpu")   # an interrupted run: the data ends early
        t.train(resume_from_checkpoint=resume)
        return model, t

    m_full, t_full = run(6, tmp_path / "a")
    assert newest_complete_checkpoint(str(tmp_path / "a")).endswith("checkpoint-6")
    m_part, _ = run(3, tmp_path / "b")
    m_res, t_res = run(6, tmp_path / "b", resume="auto")
    assert t_res.global_step == 6
    for (n, a), (_, b) in zip(m_full.named_parameters(), m_res.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), n
    os.remove(os.path.join(tmp_path, "b", "checkpoint-6", "trainer_state.json"))
    assert newest_complete_checkpoint(str(tmp_path / "b")).endswith("checkpoint-3")


def test_preference_and_grpo_trainers_step():
    cfg, model = _tiny(moe=True)
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 512, size=n) for n in (20, 24, 18, 30)]
    base = pack_documents(docs)
    pb = PreferenceBatch(base.input_ids, base.position_ids, base.labels, base.cu_seqlens, base.n_scored,
                         ref_logps=torch.full((4,), -100.0))
    args = TrainingArguments(output_dir="unused", max_steps=2, learning_rate=1e-3, optim="adamw_torch")
    t = PreferenceTrainer(model, args, [pb, pb], pref_args=PreferenceArguments(beta=0.1), device="cpu")
    assert t.train()["global_step"] == 2

    def source(i):
        return synthetic_rollouts(i, n_prompts=2, n_generations=4, vocab=512, prompt_len=(4, 8), response_len=(6, 12)) if i < 2 else None

    g = GRPOTrainer(model, TrainingArguments(output_dir="unused", max_steps=2, learning_rate=1e-3, optim="adamw_torch"),
                    source, grpo_args=GRPOArguments(num_generations=4, token_budget=64), device="cpu")
    out = g.train()
    assert out["global_step"] == 2 and all(math.isfinite(l["loss"]) for l in out["log_history"])


def test_grpo_round_is_one_optimizer_step_whatever_the_token_budget():
    """Three rounds cut into several micro-batches each: three optimizer steps, the next round's rollouts are asked
    for only after the previous round's update and weight push, and the loss scale does not depend on the cut."""
    events = []

    class Push:
        def push(self, model):
            events.append("push")

    def run(budget, loss_type):
        cfg, model = _tiny(moe=False)
        del events[:]

        def source(i):
            events.append(f"rollouts {i}")
            return synthetic_rollouts(i, n_prompts=2, n_generations=4, vocab=512, prompt_len=(4, 8), response_len=(6, 12)) if i < 3 else None

        t = GRPOTrainer(model, TrainingArguments(output_dir="unused", learning_rate=1e-3, optim="adamw_torch", logging_steps=1),
                        source, grpo_args=GRPOArguments(num_generations=4, token_budget=budget, loss_type=loss_type,
                                                        max_completion_length=12), device="cpu", weight_sync=Push())
        steps = []
        orig = t.engine.clip_and_step

        def counted_step():
            steps.append(len(events))
            events.append("step")
            orig()

        t.engine.clip_and_step = counted_step
        out = t.train()
        return out, list(events), model

    out, ev, m_small = run(40, "dapo")
    assert out["global_step"] == 3 and ev.count("step") == 3
    assert ev == ["rollouts 0", "step", "push", "rollouts 1", "step", "push", "rollouts 2", "step", "push", "rollouts 3"]
    for lt in ("dapo", "grpo", "dr_grpo"):
        a, _, ma = run(40, lt)              # 3-4 micro-batches per round
        b, _, mb = run(4096, lt)            # one micro-batch per round
        for x, y in zip(a["log_history"], b["log_history"]):
            assert x["loss"] == pytest.approx(y["loss"], rel=1e-4, abs=1e-6), lt
        for (n, p), (_, q) in zip(ma.named_parameters(), mb.named_parameters()):
            assert torch.allclose(p, q, atol=2e-5), (lt, n)


def test_world_metrics_and_small_callbacks():
    from halo_b200.callbacks.extras import EarlyStopCallback, VariableSchedulerCallback
    from halo_b200.trainers.metrics import WorldMetrics

    m = WorldMetrics()
    m.add_sum("tokens", 10)
    m.add_sum("tokens", torch.tensor(5.0))
    m.add_mean("loss", 6.0, 3)
    m.add_mean("loss", 2.0, 1)
    m.add_fraction("clipped", 1, 4)
    m.add_max("grad_norm", 2.0)
    m.add_max("grad_norm", torch.tensor(7.0))
    out = m.reduce()
    assert out == {"tokens": 15.0, "loss": 2.0, "clipped": 0.25, "grad_norm": 7.0}
    assert m.reduce() == {}
    pts = [(0, 0.1), (100, 0.5)]
    assert abs(VariableSchedulerCallback.value_at(pts, 50) - 0.3) < 1e-9 and VariableSchedulerCallback.value_at(pts, 500) == 0.5

    class T:
        class args:
            max_steps = 100
        global_step = 7

    es = EarlyStopCallback("eval_loss", patience=2)
    for v in (1.0, 0.9, 0.95, 0.97):
        es.on_log(T, {"eval_loss": v})
    assert T.args.max_steps == 7


def test_grpo_mask_stages_rank_rewards_reference_cache_and_async_source(tmp_path):
    import time

    import numpy as np

    from halo_b200.trainers.grpo import objective as ob
    from halo_b200.trainers.grpo.async_rollouts import AsyncRolloutSource
    from halo_b200.trainers.grpo.reference_cache import ReferenceCache

    traj = torch.tensor([0, 0, 0, 1, 1, 2, 2, 2])
    mask = torch.ones(8, dtype=torch.bool)
    logratio = torch.tensor([0.0, 0.1, -0.1, 2.0, 2.0, 0.0, 0.0, 6.0])
    band = ob.geometric_mean_band_mask(logratio, traj, 3, mask, 0.5, 2.0)
    assert band.tolist() == [True] * 3 + [False] * 2 + [False] * 3          # traj 1: e^2, traj 2: e^2 > 2
    low = torch.tensor([0.0, 0.1, -0.1, 2.0, 2.0, 0.0, -12.0, 6.0])
    veto = ob.raw_ratio_veto_mask(low, traj, 3, mask, veto_min=1e-4)
    assert veto.tolist() == [True] * 5 + [False] * 3                         # only traj 2 holds a ratio below 1e-4 (e^-12)
    certain = mask.clone()
    certain[6] = False                                                       # ... unless that token is not a corrected one
    assert ob.raw_ratio_veto_mask(low, traj, 3, certain, veto_min=1e-4).all()
    adv = torch.tensor([-1.0] * 3 + [1.0] * 2 + [-1.0] * 3)
    lr = torch.tensor([-0.5] * 3 + [0.5] * 2 + [0.05] * 3)                   # trainer - sampler
    opsm = ob.off_policy_sequence_mask(lr, mask, adv, traj, 3, 0.1)
    assert opsm.tolist() == [False] * 3 + [True] * 5                         # negative advantage AND |mean| > delta: traj 0 only
    assert ob.off_policy_sequence_mask(-lr, mask, adv, traj, 3, 0.1).tolist() == [False] * 3 + [True] * 5   # either direction
    r = ob.dense_rank_rewards([(1, 0), (1, 5), (0, 9), (1, 5), (2, 2), (2, 2), (2, 2), (2, 2)], 4)
    assert r.tolist() == [0.5, 1.0, 0.0, 1.0, 0.5, 0.5, 0.5, 0.5]
    c = ob.centered_logprobs(torch.tensor([-1.0]), torch.tensor([[-1.0, -3.0, -9.0]]), torch.tensor([[True, True, False]]))
    assert torch.allclose(c, torch.tensor([1.0]))

    rows = [np.arange(3, dtype=np.float32), np.zeros(0, dtype=np.float32), np.ones(5, dtype=np.float32) * -2]
    cache = ReferenceCache.build(str(tmp_path / "ref"), "k1", rows)
    assert len(cache) == 3 and cache[0].tolist() == [0, 1, 2] and cache[1].size == 0 and cache[2].sum() == -10
    assert ReferenceCache.exists(str(tmp_path / "ref"), "k1") and not ReferenceCache.exists(str(tmp_path / "ref"), "k2")

    made = []

    def generate(i, version):
        made.append((i, version))
        time.sleep(0.01)
        return None if i >= 4 else [f"round{i}@v{version}"]

    src = AsyncRolloutSource(generate, prefetch=1, max_staleness=1)
    assert src(0) == ["round0@v0"]
    src.pause()
    src.resume(3)                         # three optimizer steps later: anything produced at version <= 1 is stale
    got = src(1)
    assert got is not None and got[0].endswith("@v3") and src.discarded >= 1
    while src(0) is not None:
        pass
    src.close()


def test_efficiency_metrics_reach_the_logs(tmp_path):
    """Tokens per second and model-FLOPs utilisation come from the batches the trainer really ran."""
    import torch

    from halo_b200.callbacks.efficiency import EfficiencyCallback, model_flops_per_step
    from halo_b200.configs.arguments import TrainingArguments
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.sft import SFTTrainer

    cfg = tiny_moe_config()
    model = build_model(cfg, device="cpu", seed=0)
    batches = [synthetic_packed_batch(128, cfg.vocab_size, seed=i, lo=16, hi=64) for i in range(4)]
    eff = EfficiencyCallback(cfg, 1)
    args = TrainingArguments(output_dir=str(tmp_path / "run"), max_steps=2, optim="adamw_torch", logging_steps=1)
    trainer = SFTTrainer(model, args, iter(batches), device=torch.device("cpu"), callbacks=[eff])
    trainer.train()
    rec = trainer.log_history[-1]
    assert rec["tokens_per_s_per_gpu"] > 0 and rec["mfu"] > 0
    flops = model_flops_per_step(cfg, batches[1].cu_seqlens, batches[1].n_tokens)
    assert abs(rec["mfu"] * eff.peak * (128 / rec["tokens_per_s_per_gpu"]) / flops - 1.0) < 1e-6
    # the ranks of a tensor-parallel pair work on one row together: each accounts for half of it
    import types

    pair = EfficiencyCallback(cfg, 2)
    pair.on_batch(types.SimpleNamespace(model=types.SimpleNamespace(tensor_parallel=types.SimpleNamespace(size=2))), batches[0])
    assert pair._tokens == batches[0].n_tokens / 2 and abs(pair._flops - model_flops_per_step(cfg, batches[0].cu_seqlens, 128) / 2) < 1.0


@pytest.mark.parametrize("method,extra,arch", [("classification", "num_labels: 4\n", "Qwen3MoeForSequenceClassification"),
                                               ("embedding", "temperature: 0.1\n", "Qwen3MoeForCausalLM")])
def test_classification_and_embedding_entry_points(tmp_path, method, extra, arch):
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "c.yaml"
    cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\ndataset_format: synthetic\npacked_row_length: 256\n"
                   f"max_steps: 3\noptim: adamw_torch\noutput_dir: {tmp_path}/run\n" + extra)
    r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", method, str(cfg), "-n", "1"], cwd=root,
                       capture_output=True, text=True, timeout=240, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "step 3 " in r.stdout + r.stderr
    assert json.load(open(tmp_path / "run" / "final" / "config.json"))["architectures"] == [arch]
    if method == "embedding":
        # the pipeline description a sentence-transformers loader reads, and the embedding metrics in the log
        final = tmp_path / "run" / "final"
        modules = json.load(open(final / "modules.json"))
        assert [m["type"].rsplit(".", 1)[1] for m in modules] == ["Transformer", "Pooling", "Normalize"] and modules[0]["path"] == ""
        pool = json.load(open(final / "1_Pooling" / "config.json"))
        assert pool["pooling_mode_lasttoken"] and not pool["pooling_mode_mean_tokens"] and pool["word_embedding_dimension"] > 0
        assert json.load(open(final / "sentence_bert_config.json"))["max_seq_length"] == 256
        assert "embed/mrr" in r.stdout + r.stderr and "embed/cos_sim" in r.stdout + r.stderr


def test_embedding_pooling_and_metrics():
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.reward import embedding_metrics, last_token_states, pooled_states

    model = build_model(tiny_moe_config(), device="cpu", seed=0, gradient_checkpointing=False)
    batch = synthetic_packed_batch(96, model.cfg.vocab_size, seed=1, lo=10, hi=30)
    h = model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
    mean = pooled_states(model, batch, "mean")
    cu = [int(x) for x in batch.cu_seqlens]
    for i, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        assert torch.allclose(mean[i], h[a:b].float().mean(0), atol=1e-5)
    assert torch.equal(pooled_states(model, batch, "last_token"), last_token_states(model, batch))
    with pytest.raises(ValueError):
        pooled_states(model, batch, "cls")
    q = torch.nn.functional.normalize(torch.eye(4) + 0.01, dim=-1)
    perfect = embedding_metrics(q, q.clone(), torch.full((8,), 3.0))
    assert perfect["embed/mrr"] == 1.0 and perfect["embed/cos_sim"] > 0.999 and perfect["embed/norm"] == 3.0
    shuffled = embedding_metrics(q, q[[1, 0, 3, 2]], torch.ones(8))
    assert 0.25 <= shuffled["embed/mrr"] <= 0.5 and shuffled["embed/std"] > 0            # every positive is outranked by the query's twin


# ---- SDPG: GRPO + on-policy self-distillation from a privileged (hinted) pass of the same policy ----------------------
def test_sdpg_schedule_hint_and_pairing():
    import numpy as np

    from halo_b200.trainers.grpo.sdpg import beta_schedule, build_opd_plan, render_hint
    from halo_b200.trainers.grpo.trainer import Rollout, build_grpo_batch

    assert [round(beta_schedule(s, 10, 2.0, warmup_steps=4, decay_steps=2), 3) for s in range(10)] == \
        [0.5, 1.0, 1.5, 2.0, 2.0, 2.0, 2.0, 2.0, 1.0, 0.0]
    assert render_hint("answer: {answer}", "42") == "answer: 42" and render_hint("answer: {answer}", "  ") is None
    with pytest.raises(ValueError):
        render_hint("{solution}", "x")
    r0 = Rollout(np.array([1, 2, 3]), np.array([10, 11]), None, 1.0, teacher_prompt_ids=np.array([1, 2, 3, 7, 8]))
    r1 = Rollout(np.array([4, 5]), np.array([12, 13, 14]), None, 0.0, completion_mask=np.array([1, 0, 1]))
    adv = torch.tensor([0.7, -0.7])
    batch = build_grpo_batch([r0, r1], adv, torch.zeros(2, dtype=torch.bool))
    plan = build_opd_plan([r0, r1], batch.cu_seqlens, adv, positive_only=True)
    # student stream: [1 2 3 10 11 | 4 5 12 13 14]; teacher stream: [1 2 3 7 8 10 11 | 4 5 12 13 14]
    assert plan.student_idx.tolist() == [2, 3, 6, 8] and plan.teacher_idx.tolist() == [4, 5, 8, 10]
    assert plan.gate.tolist() == [1.0, 1.0, 0.0, 0.0]
    # the paired positions predict the same token in both streams
    for s, t in zip(plan.student_idx.tolist(), plan.teacher_idx.tolist()):
        assert batch.input_ids[s + 1] == plan.input_ids[t + 1]


def test_sdpg_adds_beta_times_gated_reverse_kl_to_the_grpo_loss():
    import numpy as np

    from halo_b200.configs.arguments import GRPOArguments, TrainingArguments
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.grpo.sdpg import SDPGTrainer
    from halo_b200.trainers.grpo.trainer import GRPOTrainer, Rollout

    torch.manual_seed(0)
    cfg = PRESETS["tiny-moe"]()
    model = build_model(cfg, device="cpu", dtype=torch.float32)
    rng = np.random.default_rng(0)
    rollouts = []
    for p in range(2):
        prompt = rng.integers(0, cfg.vocab_size, 5)
        for g in range(2):
            comp = rng.integers(0, cfg.vocab_size, 4)
            rollouts.append(Rollout(prompt, comp, None, float(g), teacher_prompt_ids=np.concatenate([prompt, rng.integers(0, cfg.vocab_size, 3)])))
    args = TrainingArguments(max_steps=4, learning_rate=1e-3, optim="adamw_torch", output_dir="/tmp/halo_b200_runs/sdpg_unit")
    gargs = GRPOArguments(num_generations=2, token_budget=4096, loss_type="dapo")
    plain = GRPOTrainer(model, args, lambda i: None, grpo_args=gargs, device=torch.device("cpu"))
    sdpg = SDPGTrainer(model, args, lambda i: None, grpo_args=gargs, device=torch.device("cpu"), sdpg_beta_base=0.5)
    (pb,) = plain.plan_round(rollouts)
    (sb,) = sdpg.plan_round(rollouts)
    base = plain.compute_loss(model, pb, None)
    total = sdpg.compute_loss(model, sb, None)
    # the term by hand: reverse KL at the completion positions of the positive-advantage rows (generation 1 of each prompt)
    with torch.no_grad():
        hs = model.hidden_states(sb.input_ids, sb.position_ids, sb.cu_seqlens).reshape(-1, cfg.hidden_size)
        ht = model.hidden_states(sb.opd.input_ids, sb.opd.position_ids, sb.opd.cu_seqlens).reshape(-1, cfg.hidden_size)
        w = model.head_weight().float()
        s = torch.log_softmax(hs[sb.opd.student_idx].float() @ w.t(), -1)
        t = torch.log_softmax(ht[sb.opd.teacher_idx].float() @ w.t(), -1)
        rkl = (s.exp() * (s - t)).sum(-1)
        want = (rkl * sb.opd.gate).sum() / sb.opd.gate.sum()
    assert sb.opd.gate.sum() == 8 and sb.opd.denominator == 8.0
    assert torch.allclose(total - base, 0.5 * want, rtol=1e-4, atol=1e-6)
    assert float(want) > 0
    # gradients reach the student only: the loss has a gradient, and a zero beta is exactly GRPO
    total.backward()
    assert all(p.grad is None or torch.isfinite(p.grad).all() for p in model.parameters())
    off = SDPGTrainer(model, args, lambda i: None, grpo_args=gargs, device=torch.device("cpu"), sdpg_beta_base=0.0)
    (ob,) = off.plan_round(rollouts)
    assert torch.equal(off.compute_loss(model, ob, None), base)


def test_hinted_source_attaches_each_rows_own_answer():
    import numpy as np

    from halo_b200.trainers.grpo.sdpg import HintedSource
    from halo_b200.trainers.grpo.trainer import Rollout

    class Source:
        mean_reward = 0.5

        def __call__(self, i):
            self.last_tasks = [{"answer": "7"}, {"answer": "7"}, {}, None]
            return [Rollout(np.array([1, 2]), np.array([3]), None, 0.0) for _ in range(4)]

    class Tok:
        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [100 + int(c) for c in text if c.isdigit()]}

    src = HintedSource(Source(), Tok(), "answer", "the answer is {answer}")
    rollouts = src(0)
    assert rollouts[0].teacher_prompt_ids.tolist() == [1, 2, 107] and rollouts[1].teacher_prompt_ids.tolist() == [1, 2, 107]
    assert rollouts[2].teacher_prompt_ids is None and rollouts[3].teacher_prompt_ids is None
    assert src.rows_without_answer == 2 and src.mean_reward == 0.5
    with pytest.raises(ValueError):
        HintedSource(Source(), Tok(), "answer", "{solution}")
