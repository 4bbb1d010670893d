"""GRPO trainers.

``GRPOTrainer`` consumes *rounds*: a round is a set of rollouts (prompt + sampled completion token
ids, the sampler's per-token log-probs, one reward per completion, grouped ``num_generations`` per
prompt). It computes group-relative advantages, packs the rows into token-budget micro-batches,
takes the importance ratios from the loss forward itself when nothing needs the old log-probs
earlier (on-policy, one iteration), and applies the clipped token objective. After the update the
weights are pushed to the rollout copy through the weight-sync group.

Rollouts come from a ``rollout_source`` callable: an offline dataset of stored rollouts, a live
engine client, or the synthetic generator used by the benchmark configuration (the trainers of
halo/trainers/grpo/offline/*, online.py and environmental/*)."""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from halo_b200.configs.arguments import GRPOArguments
from halo_b200.data.packing import PackedBatch, pack_documents
from halo_b200.trainers.base import Trainer
from halo_b200.trainers.grpo import advantages as adv_mod
from halo_b200.trainers.grpo import microbatch, objective


@dataclass
class Rollout:
    prompt_ids: np.ndarray
    completion_ids: np.ndarray
    sampler_logprobs: np.ndarray | None   # per completion token; None = treat as on-policy
    reward: float
    completion_mask: np.ndarray | None = None   # 1 on tokens the policy produced, 0 on environment tokens in between; None = all 1
    routing: np.ndarray | None = None           # [moe layers, prompt + completion - 1, top_k]: the sampler's experts per token
    routing_layers: list | None = None          # the decoder-layer index of every row of ``routing``
    teacher_prompt_ids: np.ndarray | None = None  # prompt + privileged hint, for the self-distillation term (None = plain prompt)


@dataclass
class GRPOBatch(PackedBatch):
    advantages: torch.Tensor = None       # [T] advantage of the row each token belongs to
    old_logprobs: torch.Tensor = None     # [T] sampler log-probs aligned with labels (0 where unknown)
    has_old: bool = False
    degenerate: torch.Tensor = None       # [T] bool: token belongs to a zero-spread group
    seq_lengths: torch.Tensor = None      # [n_rows] completion lengths
    attention_mask: torch.Tensor = None   # [T, T] bool under tree packing (prompts stored once per group)
    replay_routing: dict = None           # {layer index: [T, top_k] int32, -1 = unknown}: the sampler's routing to replay
    traj_ids: torch.Tensor = None         # [T] index (within this batch) of the row each token belongs to
    counted_tokens: list = None           # per row: policy-produced completion tokens (host side)
    denominator: float = 0.0              # the whole round's loss denominator over every micro-batch and rank (0 = not set)

    def to(self, device, non_blocking: bool = True):
        b = PackedBatch.to(self, device, non_blocking)
        mv = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)  # noqa: E731
        out = GRPOBatch(b.input_ids, b.position_ids, b.labels, b.cu_seqlens, b.n_scored, mv(self.advantages),
                        mv(self.old_logprobs), self.has_old, mv(self.degenerate), mv(self.seq_lengths), mv(self.attention_mask),
                        None if self.replay_routing is None else {k: mv(v) for k, v in self.replay_routing.items()},
                        mv(self.traj_ids), self.counted_tokens, self.denominator)
        out.opd = getattr(self, "opd", None)
        return out


def build_grpo_batch(rollouts: list[Rollout], adv: torch.Tensor, degenerate: torch.Tensor) -> GRPOBatch:
    docs, masks = [], []
    for r in rollouts:
        docs.append(np.concatenate([r.prompt_ids, r.completion_ids]))
        own = np.ones(len(r.completion_ids), bool) if r.completion_mask is None else np.asarray(r.completion_mask, bool)
        masks.append(np.concatenate([np.zeros(len(r.prompt_ids), bool), own]))
    base = pack_documents(docs, label_masks=masks)
    T = base.n_tokens
    a = torch.zeros(T)
    old = torch.zeros(T)
    deg = torch.zeros(T, dtype=torch.bool)
    traj = torch.zeros(T, dtype=torch.int64)
    has_old = all(r.sampler_logprobs is not None for r in rollouts)
    for i, r in enumerate(rollouts):
        s, e = int(base.cu_seqlens[i]), int(base.cu_seqlens[i + 1])
        a[s:e] = float(adv[i])
        traj[s:e] = i
        deg[s:e] = bool(degenerate[i])
        if has_old:
            # label at position t scores token t+1: completion token j sits at label index len(prompt) + j - 1
            p = len(r.prompt_ids)
            old[s + p - 1:s + p - 1 + len(r.completion_ids)] = torch.from_numpy(np.asarray(r.sampler_logprobs, np.float32))
    replay = None
    if all(r.routing is not None for r in rollouts):
        layers, k = rollouts[0].routing_layers, rollouts[0].routing.shape[-1]
        replay = {li: torch.full((T, k), -1, dtype=torch.int32) for li in layers}
        for i, r in enumerate(rollouts):
            s = int(base.cu_seqlens[i])
            n = min(r.routing.shape[1], len(r.prompt_ids) + len(r.completion_ids))
            for row, li in enumerate(layers):
                replay[li][s:s + n] = torch.from_numpy(r.routing[row, :n].astype(np.int32))
    batch = GRPOBatch(base.input_ids, base.position_ids, base.labels, base.cu_seqlens, base.n_scored, a, old, has_old,
                      deg, torch.tensor([len(r.completion_ids) for r in rollouts], dtype=torch.float32), None, replay,
                      traj, [counted_completion_tokens(r) for r in rollouts])
    batch.rollouts = rollouts           # host side only: plans layered on the batch (self-distillation) read the rows
    return batch


def counted_completion_tokens(r: Rollout) -> int:
    """Completion tokens of a rollout that the policy itself produced (environment tokens in between do not count)."""
    return int(len(r.completion_ids) if r.completion_mask is None else np.asarray(r.completion_mask, bool).sum())


def filler_batch() -> GRPOBatch:
    """A micro-batch that scores nothing: three tokens, every label ignored. A rank that has fewer rows than the
    world has micro-steps runs these in the empty slots, so that it still enters every collective of the step (the
    normaliser reduction, expert dispatch, gradient reduction) and adds exactly zero to the loss and the gradients."""
    r = Rollout(np.zeros(2, np.int64), np.zeros(1, np.int64), None, 0.0, completion_mask=np.zeros(1, bool))
    return build_grpo_batch([r], torch.zeros(1), torch.ones(1, dtype=torch.bool))


def build_grpo_tree_batch(rollouts: list[Rollout], adv: torch.Tensor, degenerate: torch.Tensor, group_size: int) -> GRPOBatch:
    """The same round with every prompt stored once: the ``group_size`` completions of a prompt are branches of one tree
    (:mod:`halo_b200.data.tree_layout`). ``rollouts`` hold the generations of a prompt contiguously."""
    from halo_b200.data.tree_layout import pack_trees

    if len(rollouts) % group_size:
        raise ValueError(f"{len(rollouts)} rollouts do not split into groups of {group_size}")
    groups, masks = [], []
    for g0 in range(0, len(rollouts), group_size):
        members = rollouts[g0:g0 + group_size]
        if any(not np.array_equal(m.prompt_ids, members[0].prompt_ids) for m in members):
            raise ValueError("tree packing needs the generations of a prompt to sit together")
        groups.append((members[0].prompt_ids, [m.completion_ids for m in members]))
        masks.append([np.ones(len(m.completion_ids), bool) if m.completion_mask is None else np.asarray(m.completion_mask, bool)
                      for m in members])
    tree = pack_trees(groups, masks)
    T = tree.input_ids.numel()
    a, old, deg = torch.zeros(T), torch.zeros(T), torch.zeros(T, dtype=torch.bool)
    traj = torch.zeros(T, dtype=torch.int64)
    has_old = all(r.sampler_logprobs is not None for r in rollouts)
    i = 0
    for own in tree.branch_slices:
        for start, stop in own:
            r = rollouts[i]
            lo, hi = start - 1, stop - 1                  # the labels that score this branch's completion tokens
            a[lo:hi] = float(adv[i])
            traj[lo:hi] = i
            deg[lo:hi] = bool(degenerate[i])
            if has_old:
                old[lo:hi] = torch.from_numpy(np.asarray(r.sampler_logprobs, np.float32))
            i += 1
    n_scored = int((tree.labels != -100).sum())
    return GRPOBatch(tree.input_ids, tree.position_ids, tree.labels, tree.cu_seqlens, n_scored, a, old, has_old, deg,
                     torch.tensor([len(r.completion_ids) for r in rollouts], dtype=torch.float32), tree.allowed, None,
                     traj, [counted_completion_tokens(r) for r in rollouts])


class GRPOTrainer(Trainer):
    def __init__(self, model, args, rollout_source, grpo_args: GRPOArguments | None = None, ref_model=None,
                 weight_sync=None, **kw):
        self.grpo = grpo_args or GRPOArguments()
        self.rollout_source = rollout_source
        self.ref_model = ref_model
        self.weight_sync = weight_sync
        self.rounds_done = 0
        self.zero_gradient_rounds = 0
        super().__init__(model, args, train_batches=self._rounds, **kw)

    # ---- rounds -> micro-batches ---------------------------------------------------------------
    def _world_max(self, n: int) -> int:
        if self.parallel is None:
            return n
        import torch.distributed as dist

        t = torch.tensor([n], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.parallel.dp_group)
        return int(t.item())

    def _world_sum(self, x: float) -> float:
        if self.parallel is None:
            return x
        import torch.distributed as dist

        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, group=self.parallel.dp_group)
        return float(t.item())

    def plan_round(self, rollouts: list[Rollout]) -> list[GRPOBatch]:
        """The micro-batches of one round = one optimizer step. Every rank returns the same number of them (slots a
        rank cannot fill hold a filler batch that scores nothing), and each carries the ROUND's denominator: this
        rank's share by ``loss_type``, summed over the data-parallel ranks."""
        g = self.grpo
        rewards = torch.tensor([r.reward for r in rollouts], dtype=torch.float32)
        adv, degenerate = adv_mod.group_advantages(rewards, g.num_generations, g.scale_rewards, g.std_floor)
        if bool(degenerate.all()):
            self.zero_gradient_rounds += 1
            if g.zero_gradient_round_limit and self.zero_gradient_rounds >= g.zero_gradient_round_limit:
                raise RuntimeError(f"{self.zero_gradient_rounds} rounds in a row carried no learning signal")
        else:
            self.zero_gradient_rounds = 0
        share = objective.round_denominator(g.loss_type, [counted_completion_tokens(r) for r in rollouts],
                                            [bool(d) for d in degenerate], g.max_completion_length)
        denominator = max(self._world_sum(share), 1.0)
        out = []
        world_max = self._world_max if self.parallel else None
        if getattr(g, "tree_packing", False):
            G = g.num_generations
            group_len = [len(rollouts[i].prompt_ids) - 1 + sum(1 + len(r.completion_ids) for r in rollouts[i:i + G])
                         for i in range(0, len(rollouts), G)]
            for b in microbatch.plan_microbatches(group_len, g.token_budget, world_max):
                if not b:
                    out.append(filler_batch())
                    continue
                idx = [i for gi in sorted(b) for i in range(gi * G, (gi + 1) * G)]
                out.append(build_grpo_tree_batch([rollouts[i] for i in idx], adv[idx], degenerate[idx], G))
        else:
            lengths = [len(r.prompt_ids) + len(r.completion_ids) for r in rollouts]
            for b in microbatch.plan_microbatches(lengths, g.token_budget, world_max):
                out.append(build_grpo_batch([rollouts[i] for i in b], adv[b], degenerate[b]) if b else filler_batch())
        for b in out:
            b.denominator = denominator
        return out

    def _rounds(self):
        """One list of micro-batches per round: the trainer loop runs a list as exactly one optimizer step, so the
        next round's rollouts are requested only after this round's update (and weight push) has happened."""
        while True:
            rollouts = self._shared_round(self.rounds_done)
            if rollouts is None:
                return
            batches = self.plan_round(rollouts)
            yield [b.pin() if torch.cuda.is_available() else b for b in batches]
            self.rounds_done += 1

    def _sibling_group(self):
        """The group whose ranks hold slices of ONE model replica (tensor parallel, or expert tensor parallel): they run
        collectives inside the forward, so they must train on identical rows."""
        tp = getattr(self.model, "tensor_parallel", None)
        etp = getattr(self.model, "expert_tensor_parallel", None)
        sliced = tp if tp is not None else etp
        return getattr(sliced, "group", None)

    def _shared_round(self, index: int):
        """This round's rollouts. Under tensor / expert tensor parallelism only the group's first rank asks the source;
        its rollouts (or its end-of-data) are broadcast to the siblings: independently sampled rounds would differ in
        row count and length, and the siblings' collectives would wait for each other for ever."""
        group = self._sibling_group()
        if group is None:
            return self.rollout_source(index)
        from halo_b200.runtime.collectives import share_from_leader

        return share_from_leader(lambda: self.rollout_source(index), group)

    def skip_consumed(self, it):
        """A resumed run continues with round ``global_step``: one round is one optimizer step, and rounds the
        interrupted run already trained on are not requested again."""
        self.rounds_done = self.global_step
        return it

    # ---- objective -----------------------------------------------------------------------------
    def compute_loss(self, model, batch: GRPOBatch, normalizer):
        g = self.grpo
        ctx = None
        replay = batch.replay_routing if getattr(g, "routing_replay", False) else None
        if batch.attention_mask is not None or replay is not None:
            ctx = model.make_context(batch.position_ids.reshape(-1), batch.cu_seqlens, replay_topk=replay)
            ctx.attention_mask = batch.attention_mask
        logp, _ = model.token_logprobs(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels, ctx=ctx)
        mask = batch.labels.reshape(-1) != -100
        # on-policy single iteration: the old log-probs are this forward's own (detached) values
        old = batch.old_logprobs if (batch.has_old and g.num_iterations > 1) else logp.detach()
        is_w = None
        if batch.has_old:
            is_w = objective.importance_weights(logp, batch.old_logprobs, mask, g.importance_clip_max)
            if g.trust_region_mask_fraction < 1.0:
                # the breaker: too many tokens at the importance cap means the sampler and the trainer have drifted
                # apart; the whole round's update is skipped on every rank (the flag stays on the device)
                over = (objective.capped_fraction(is_w, mask, g.importance_clip_max) > g.trust_region_mask_fraction).to(torch.int32)
                prev = self.engine.skip_request
                self.engine.skip_request = over if prev is None else torch.maximum(prev, over)
            is_w = self._apply_mask_stages(is_w, logp, batch, mask)
        ref = None
        if g.grpo_beta and self.ref_model is not None:
            with torch.no_grad():
                ref, _ = self.ref_model.token_logprobs(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
        tok_w = None
        if g.loss_type == "grpo":
            # the per-sequence mean: every counted token weighs 1 / (counted tokens of its row)
            per_row = torch.tensor([1.0 / max(n, 1) for n in batch.counted_tokens], dtype=torch.float32, device=logp.device)
            tok_w = per_row[batch.traj_ids.reshape(-1)]
        elif g.loss_type in ("dapo", "bnpo"):
            tok_w = (~batch.degenerate.reshape(-1)).to(torch.float32)      # rows without a signal leave the numerator too
        num, _ = objective.grpo_token_loss(logp, old, batch.advantages, mask, g.epsilon, g.epsilon_high, g.grpo_beta,
                                           ref, is_w, tok_w)
        # one denominator for the whole round (all micro-batches, all data-parallel ranks): gradients are SUMMED over
        # both, so the loss scale changes neither with the token budget nor with the data-parallel width
        if batch.denominator > 0:
            return num / batch.denominator
        denom = objective.normalizer(g.loss_type, mask, batch.seq_lengths, g.max_completion_length, batch.degenerate)
        return num / denom

    def _apply_mask_stages(self, is_w, logp, batch: GRPOBatch, mask):
        """The optional trajectory masks (all off by default): a masked trajectory's importance weight becomes 0, which
        removes its surrogate term and leaves the denominator and the KL anchor in place."""
        g = self.grpo
        if g.is_geo_band_min is None and g.is_veto_min is None and g.opsm_delta is None:
            return is_w
        traj = batch.traj_ids.reshape(-1)
        n_traj = len(batch.counted_tokens)
        corrected = objective.corrected_tokens(batch.old_logprobs, mask)
        logratio = (logp.detach() - batch.old_logprobs) * corrected
        keep = torch.ones_like(mask)
        if g.is_geo_band_min is not None:
            keep &= objective.geometric_mean_band_mask(logratio, traj, n_traj, corrected, g.is_geo_band_min, g.is_geo_band_max)
        if g.is_veto_min is not None:
            keep &= objective.raw_ratio_veto_mask(logratio, traj, n_traj, corrected, g.is_veto_min)
        if g.opsm_delta is not None:
            keep &= objective.off_policy_sequence_mask(logratio, corrected, batch.advantages, traj, n_traj, g.opsm_delta)
        return torch.where(keep, is_w, torch.zeros_like(is_w))

    def extra_logs(self) -> dict:
        out = {}
        src = self.rollout_source
        if hasattr(src, "mean_reward"):
            out["rollout_reward"] = float(src.mean_reward)
        if hasattr(src, "last_version"):
            out["rollout_version"] = int(src.last_version)
            out["rollout_wait_seconds"] = float(src.waited_seconds)
        return out

    # ---- weight push ---------------------------------------------------------------------------
    def after_optimizer_step(self):
        if self.weight_sync is not None and self.global_step % max(1, self.grpo.sync_weights_every) == 0:
            self.weight_sync.push(self.model)


def synthetic_rollouts(round_index: int, n_prompts: int = 64, n_generations: int = 8, vocab: int = 151936,
                       prompt_len=(128, 1024), response_len=(256, 4096), seed: int = 0) -> list[Rollout]:
    """Random token ids, N(0,1) rewards (the synthetic rollouts of the asynchronous-GRPO benchmark)."""
    rng = np.random.default_rng(seed * 100003 + round_index)
    out = []
    for _ in range(n_prompts):
        prompt = rng.integers(0, vocab, size=int(rng.integers(prompt_len[0], prompt_len[1] + 1)))
        for _ in range(n_generations):
            comp = rng.integers(0, vocab, size=int(rng.integers(response_len[0], response_len[1] + 1)))
            out.append(Rollout(prompt, comp, None, float(rng.normal())))
    return out
